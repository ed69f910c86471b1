"""Gibalorn: config.json -> typed configuration -> :class:`ModelSpec`.

A decoder-only model whose config.json lists its layers one by one (``layers``: ``type``, the mixer's sizes under
``mixer``, the feed-forward under ``mlp`` or null) and may run a stretch of them several times (``loop``: layers
``start .. stop - 1`` run ``times`` times in a row with the same weights, every pass with caches and states of its own,
and before every pass but the first the embedding's output is added to the residual stream).  Pre-norm layers with plain
RMS norms; three kinds of mixer:

* ``attention``: grouped-query attention without a value projection (a token's value is its key before the turn),
  rotate-half rotation of the first ``rot.dims`` entries of a head, ``scale`` from the config, and a softmax whose
  denominator holds one more term of score 0;
* ``latent_attention``: queries through a normed latent, keys and values as up-projections of a cached normed latent, a
  turned key part shared by all heads (interleaved pairing), an ordinary softmax, and a sigmoid output gate;
* ``mamba2``: a selective state-space layer with a short causal convolution and a gated, grouped norm.

The feed-forward is a routed one: sigmoid scores, the ``top`` largest chosen and used unrenormalised as weights on the
experts' *inputs*; an expert is ``down(max(up x, 0)^2)``.  The head is a tensor of its own.

Tensor names: ``embed``, ``head``, ``final.norm``, and per layer i ``l<i>.norm1``, ``l<i>.norm2``, ``l<i>.mix.*``,
``l<i>.mlp.*``.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Mapping, Optional, Tuple

from ..config.registry import ConfigError, register_architecture
from ..config.spec import LayerCall, LayerSpec, ModelSpec, PartSpec

MIXER_TYPES = ("attention", "latent_attention", "mamba2")
# the framework's context limit when config.json names none: the design has no learned positions
DEFAULT_MAX_POSITIONS = 1 << 15


@dataclass(frozen=True)
class GibalornRotation:
    base: float
    dims: int


@dataclass(frozen=True)
class GibalornLayer:
    type: str
    mixer: Mapping[str, Any]              # the mixer's sizes, checked
    rot: Optional[GibalornRotation]
    experts: int = 0                      # 0: no feed-forward
    top: int = 0
    ff: int = 0


@dataclass(frozen=True)
class GibalornConfig:
    vocab: int
    width: int
    eps: float
    layers: Tuple[GibalornLayer, ...]
    loop_start: int
    loop_stop: int
    loop_times: int
    max_positions: int
    raw: Mapping[str, Any]

    def to_json_dict(self) -> dict:
        return dict(self.raw)

    def run_order(self) -> Tuple[Tuple[int, bool], ...]:
        """(layer, is the first layer of a pass after the first) for every call, in order."""
        out = [(i, False) for i in range(self.loop_start)]
        for rep in range(self.loop_times):
            out.extend((i, rep > 0 and i == self.loop_start) for i in range(self.loop_start, self.loop_stop))
        out.extend((i, False) for i in range(self.loop_stop, len(self.layers)))
        return tuple(out)


def _int(obj: Mapping[str, Any], key: str, where: str) -> int:
    v = obj.get(key)
    if isinstance(v, bool) or not isinstance(v, int) or v <= 0:
        raise ConfigError(f"config.json: {where}'{key}' must be a positive integer, got {v!r}")
    return v


def _num(obj: Mapping[str, Any], key: str, where: str) -> float:
    v = obj.get(key)
    if isinstance(v, bool) or not isinstance(v, (int, float)):
        raise ConfigError(f"config.json: {where}'{key}' must be a number, got {v!r}")
    return float(v)


def _rotation(m: Mapping[str, Any], where: str, limit: int) -> GibalornRotation:
    rot = m.get("rot")
    if not isinstance(rot, Mapping):
        raise ConfigError(f"config.json: {where}rot must be an object with 'base' and 'dims'")
    base, dims = _num(rot, "base", where + "rot."), _int(rot, "dims", where + "rot.")
    if not base > 0.0 or dims % 2 or dims > limit:
        raise ConfigError(f"config.json: {where}rot: base={base} must be positive and dims={dims} even and at most {limit}")
    return GibalornRotation(base, dims)


def parse_gibalorn_config(raw: Mapping[str, Any]) -> GibalornConfig:
    missing = [k for k in ("vocab", "width", "layers", "norm") if k not in raw]
    if missing:
        raise ConfigError("config.json: missing required key(s): " + ", ".join(missing))
    if not isinstance(raw["layers"], list) or not raw["layers"]:
        raise ConfigError("config.json: 'layers' must be a list with at least one layer")
    if not isinstance(raw["norm"], Mapping):
        raise ConfigError("config.json: 'norm' must be an object with 'eps'")
    eps = _num(raw["norm"], "eps", "norm.")
    if not eps > 0.0:
        raise ConfigError(f"config.json: norm.eps={eps} must be positive")
    layers = []
    for i, entry in enumerate(raw["layers"]):
        where = f"layers[{i}]."
        if not isinstance(entry, Mapping) or not isinstance(entry.get("mixer"), Mapping):
            raise ConfigError(f"config.json: {where}mixer must be an object")
        kind, m, mw = entry.get("type"), entry["mixer"], where + "mixer."
        rot = None
        if kind == "attention":
            sizes = {k: _int(m, k, mw) for k in ("heads", "kv_heads", "dim")}
            sizes["vdim"] = _int(m, "vdim", mw) if "vdim" in m else sizes["dim"]
            if sizes["heads"] % sizes["kv_heads"]:
                raise ConfigError(f"config.json: {mw}heads={sizes['heads']} is no multiple of kv_heads={sizes['kv_heads']}")
            if sizes["vdim"] != sizes["dim"]:
                raise ConfigError(f"config.json: {mw}vdim={sizes['vdim']} differs from dim={sizes['dim']}, but the values are the keys")
            sizes["scale"] = _num(m, "scale", mw)
            rot = _rotation(m, mw, sizes["dim"])
        elif kind == "latent_attention":
            sizes = {k: _int(m, k, mw) for k in ("heads", "dim", "rot_dim", "vdim", "kv_rank", "q_rank")}
            sizes["scale"] = _num(m, "scale", mw)
            rot = _rotation(m, mw, sizes["rot_dim"])
        elif kind == "mamba2":
            sizes = {k: _int(m, k, mw) for k in ("heads", "vdim", "state", "groups", "conv", "norm_groups")}
            if sizes["heads"] % sizes["groups"]:
                raise ConfigError(f"config.json: {mw}heads={sizes['heads']} is no multiple of groups={sizes['groups']}")
            if (sizes["heads"] * sizes["vdim"]) % sizes["norm_groups"]:
                raise ConfigError(f"config.json: {mw}norm_groups={sizes['norm_groups']} does not divide heads * vdim")
        else:
            raise ConfigError(f"config.json: {where}type={kind!r} is not a mixer of this design ({', '.join(MIXER_TYPES)})")
        f = entry.get("mlp")
        experts = top = ff = 0
        if f is not None:
            if not isinstance(f, Mapping):
                raise ConfigError(f"config.json: {where}mlp must be an object or null")
            if f.get("kind", "moe") != "moe":
                raise ConfigError(f"config.json: {where}mlp.kind={f.get('kind')!r} is not 'moe'")
            ex, router = f.get("expert"), f.get("router")
            if not isinstance(ex, Mapping) or not isinstance(router, Mapping):
                raise ConfigError(f"config.json: {where}mlp needs 'expert' and 'router' objects")
            experts, top = _int(router, "experts", where + "mlp.router."), _int(router, "top", where + "mlp.router.")
            ff = _int(ex, "ff", where + "mlp.expert.")
            if top > experts:
                raise ConfigError(f"config.json: {where}mlp.router.top={top} exceeds experts={experts}")
        layers.append(GibalornLayer(kind, sizes, rot, experts, top, ff))
    start = stop = 0
    times = 1
    loop = raw.get("loop")
    if loop is not None:
        if not isinstance(loop, Mapping):
            raise ConfigError("config.json: 'loop' must be an object with 'start', 'stop' and 'times', or null")
        for k in ("start", "stop"):
            v = loop.get(k)
            if isinstance(v, bool) or not isinstance(v, int) or not 0 <= v <= len(layers):
                raise ConfigError(f"config.json: loop.{k}={v!r} must lie in 0 .. {len(layers)}")
        start, stop, times = loop["start"], loop["stop"], _int(loop, "times", "loop.")
        if stop < start:
            raise ConfigError(f"config.json: loop.stop={stop} lies before loop.start={start}")
    max_positions = _int(raw, "max_positions", "") if "max_positions" in raw else DEFAULT_MAX_POSITIONS
    return GibalornConfig(vocab=_int(raw, "vocab", ""), width=_int(raw, "width", ""), eps=eps, layers=tuple(layers),
                          loop_start=start, loop_stop=stop, loop_times=times, max_positions=max_positions, raw=dict(raw))


def build_gibalorn_spec(cfg: GibalornConfig) -> ModelSpec:
    def norm(name: str) -> PartSpec:
        return PartSpec("rmsnorm", {"size": cfg.width, "eps": cfg.eps, "name": name})

    layers = []
    for layer in cfg.layers:
        m = layer.mixer
        if layer.type == "attention":
            mixer = PartSpec("attention", {
                "hidden_size": cfg.width, "num_heads": m["heads"], "num_kv_heads": m["kv_heads"], "head_dim": m["dim"],
                "position": PartSpec("rope_span", {"head_dim": m["dim"], "dims": layer.rot.dims, "theta": layer.rot.base,
                                                   "interleaved": False}),
                "qkv_bias": False, "scale": m["scale"], "value_from_key": True, "unit_sink": True,
                "names": {"q": "q", "k": "k", "o": "o"}})
        elif layer.type == "latent_attention":
            mixer = PartSpec("latent_attention", {
                "hidden_size": cfg.width, "num_heads": m["heads"], "qk_dim": m["dim"], "v_dim": m["vdim"], "rank": m["kv_rank"],
                "eps": cfg.eps, "scale": m["scale"], "window": None, "sinks": False, "rot_dim": m["rot_dim"],
                "rot_dims": layer.rot.dims, "rot_base": layer.rot.base, "rot_interleaved": True, "q_rank": m["q_rank"],
                "out_gate": True})
        else:
            mixer = PartSpec("mamba2", {
                "hidden_size": cfg.width, "heads": m["heads"], "vdim": m["vdim"], "state": m["state"], "groups": m["groups"],
                "conv": m["conv"], "norm_groups": m["norm_groups"], "eps": cfg.eps})
        ffn, norms = None, {"norm1": norm("norm1")}
        if layer.experts:
            norms["norm2"] = norm("norm2")
            ffn = PartSpec("routed_experts", {
                "hidden_size": cfg.width, "intermediate_size": layer.ff, "experts": layer.experts, "top": layer.top,
                "router_bias": False, "activation": "relu2", "score": "sigmoid", "weight_on": "input"})
        layers.append(LayerSpec(block="pre_norm", mixer=mixer, ffn=ffn, norms=norms,
                                prefixes={"mixer": "mix.", "ffn": "mlp.", "norm1": "", "norm2": ""}))
    schedule = tuple(LayerCall(i, add_embedding=again) for i, again in cfg.run_order())
    return ModelSpec(
        architecture="Gibalorn", vocab_size=cfg.vocab, hidden_size=cfg.width, layers=tuple(layers), schedule=schedule,
        final_norm=norm("norm"), tie_word_embeddings=False, max_position_embeddings=cfg.max_positions,
        layer_prefix="l{i}.", embed_name="embed", final_norm_prefix="final.", head_name="head")


GIBALORN = register_architecture("Gibalorn", model_types=("gibalorn",), parse=parse_gibalorn_config,
                                 build_spec=build_gibalorn_spec, kernel_libraries=("rowwise", "moe", "ssm"))
