"""Baselix: config.json -> typed configuration -> :class:`ModelSpec`.

A decoder-only model whose config.json lists its layers one by one.  Token embedding plus a learned absolute position
table; pre-norm layers whose branch outputs enter the residual stream times ``residual_mult``; RMS norms whose weights
are stored around zero (factor ``1 + w``); every mixer is latent attention without a position rule, with a sliding
window (``mask.size``) and a sink logit per head, and a layer with ``kv_from: j`` has no down-projection of its own
but reads the latents layer j caches; a layer's feed-forward is dense (squared ReLU), routed (experts of a clamped,
sigmoid-gated form plus a shared one) or absent; the head is the embedding table, and the logits are capped by
``logit_softcap * tanh(logits / logit_softcap)``.

The constants the design fixes, not config.json: the gate's slope 1.702 and the ``+ 1`` on the up half of an expert.
Tensor names: ``embed``, ``pos``, ``final.norm``, and per layer i ``l<i>.norm1``, ``l<i>.norm2``, ``l<i>.mix.*``,
``l<i>.mlp.*``.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Mapping, Optional, Tuple

from ..config.registry import ConfigError, register_architecture
from ..config.spec import LayerCall, LayerSpec, ModelSpec, PartSpec

EXPERT_GATE_SLOPE = 1.702
EXPERT_UP_OFFSET = 1.0


@dataclass(frozen=True)
class BaselixMixer:
    heads: int
    dim: int
    vdim: int
    kv_rank: int
    scale: float
    window: Optional[int]
    kv_from: Optional[int]


@dataclass(frozen=True)
class BaselixFeedForward:
    kind: str                            # "dense" or "moe"
    ff: int                              # dense: the inner width; moe: an expert's
    limit: Optional[float] = None
    experts: int = 0
    top: int = 0
    shared_ff: Optional[int] = None
    shared_limit: Optional[float] = None


@dataclass(frozen=True)
class BaselixLayer:
    mixer: BaselixMixer
    mlp: Optional[BaselixFeedForward]


@dataclass(frozen=True)
class BaselixConfig:
    vocab: int
    width: int
    max_positions: int
    layers: Tuple[BaselixLayer, ...]
    eps: float
    residual_mult: float
    logit_softcap: Optional[float]
    raw: Mapping[str, Any]

    def to_json_dict(self) -> dict:
        return dict(self.raw)


def _int(obj: Mapping[str, Any], key: str, where: str) -> int:
    v = obj.get(key)
    if isinstance(v, bool) or not isinstance(v, int) or v <= 0:
        raise ConfigError(f"config.json: {where}'{key}' must be a positive integer, got {v!r}")
    return v


def _num(obj: Mapping[str, Any], key: str, where: str, default=None) -> float:
    v = obj.get(key, default)
    if isinstance(v, bool) or not isinstance(v, (int, float)):
        raise ConfigError(f"config.json: {where}'{key}' must be a number, got {v!r}")
    return float(v)


def _limit(obj: Mapping[str, Any], where: str) -> Optional[float]:
    if obj.get("limit") is None:
        return None
    v = _num(obj, "limit", where)
    if not v > 0.0:
        raise ConfigError(f"config.json: {where}'limit' must be positive, got {v!r}")
    return v


def parse_baselix_config(raw: Mapping[str, Any]) -> BaselixConfig:
    missing = [k for k in ("vocab", "width", "max_positions", "layers", "norm") if k not in raw]
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
        kind = entry.get("type")
        if kind != "latent_attention":
            raise ConfigError(f"config.json: {where}type={kind!r} is not a mixer of this design (latent_attention)")
        m = entry["mixer"]
        mask = m.get("mask")
        window = None
        if mask is not None:
            if not isinstance(mask, Mapping):
                raise ConfigError(f"config.json: {where}mixer.mask must be an object with 'size'")
            window = _int(mask, "size", where + "mixer.mask.")
        kv_from = m.get("kv_from")
        if kv_from is not None:
            if isinstance(kv_from, bool) or not isinstance(kv_from, int) or not 0 <= kv_from < i:
                raise ConfigError(f"config.json: {where}mixer.kv_from={kv_from!r} must name an earlier layer")
            if layers[kv_from].mixer.kv_from is not None:
                raise ConfigError(f"config.json: {where}mixer.kv_from={kv_from} names a layer that has no latent of its own")
        mixer = BaselixMixer(heads=_int(m, "heads", where + "mixer."), dim=_int(m, "dim", where + "mixer."),
                             vdim=_int(m, "vdim", where + "mixer."), kv_rank=_int(m, "kv_rank", where + "mixer."),
                             scale=_num(m, "scale", where + "mixer.", default=float(_int(m, "dim", where + "mixer.")) ** -0.5),
                             window=window, kv_from=kv_from)
        if kv_from is not None and layers[kv_from].mixer.kv_rank != mixer.kv_rank:
            raise ConfigError(f"config.json: {where}mixer.kv_rank={mixer.kv_rank} differs from layer {kv_from}'s "
                              f"{layers[kv_from].mixer.kv_rank}, whose latents it reads")
        f = entry.get("mlp")
        mlp = None
        if f is not None:
            if not isinstance(f, Mapping):
                raise ConfigError(f"config.json: {where}mlp must be an object or null")
            if f.get("kind") == "dense":
                mlp = BaselixFeedForward("dense", _int(f, "ff", where + "mlp."))
            elif f.get("kind") == "moe":
                ex, router = f.get("expert"), f.get("router")
                if not isinstance(ex, Mapping) or not isinstance(router, Mapping):
                    raise ConfigError(f"config.json: {where}mlp needs 'expert' and 'router' objects")
                experts, top = _int(router, "experts", where + "mlp.router."), _int(router, "top", where + "mlp.router.")
                if top > experts:
                    raise ConfigError(f"config.json: {where}mlp.router.top={top} exceeds experts={experts}")
                sh = f.get("shared")
                if sh is not None and not isinstance(sh, Mapping):
                    raise ConfigError(f"config.json: {where}mlp.shared must be an object or null")
                mlp = BaselixFeedForward("moe", _int(ex, "ff", where + "mlp.expert."), _limit(ex, where + "mlp.expert."),
                                         experts, top,
                                         _int(sh, "ff", where + "mlp.shared.") if sh is not None else None,
                                         _limit(sh, where + "mlp.shared.") if sh is not None else None)
            else:
                raise ConfigError(f"config.json: {where}mlp.kind={f.get('kind')!r} is not 'dense' or 'moe'")
        layers.append(BaselixLayer(mixer, mlp))
    cap = raw.get("logit_softcap")
    if cap is not None:
        cap = _num(raw, "logit_softcap", "")
        if not cap > 0.0:
            raise ConfigError(f"config.json: logit_softcap={cap} must be positive")
    return BaselixConfig(vocab=_int(raw, "vocab", ""), width=_int(raw, "width", ""),
                         max_positions=_int(raw, "max_positions", ""), layers=tuple(layers), eps=eps,
                         residual_mult=_num(raw, "residual_mult", "", default=1.0), logit_softcap=cap, raw=dict(raw))


def build_baselix_spec(cfg: BaselixConfig) -> ModelSpec:
    def norm(name: str) -> PartSpec:
        return PartSpec("rmsnorm", {"size": cfg.width, "eps": cfg.eps, "name": name, "unit_offset": True})

    # the latents of a layer serve every layer that names it: its cache keeps what the widest of their windows needs
    users = {i: [i] for i, layer in enumerate(cfg.layers) if layer.mixer.kv_from is None}
    for i, layer in enumerate(cfg.layers):
        if layer.mixer.kv_from is not None:
            users[layer.mixer.kv_from].append(i)
    cache_window = {}
    for owner, group in users.items():
        windows = [cfg.layers[i].mixer.window for i in group]
        keep = None if any(w is None for w in windows) else max(windows)
        for i in group:
            cache_window[i] = keep

    layers, schedule = [], []
    for i, layer in enumerate(cfg.layers):
        m = layer.mixer
        mixer = PartSpec("latent_attention", {
            "hidden_size": cfg.width, "num_heads": m.heads, "qk_dim": m.dim, "v_dim": m.vdim, "rank": m.kv_rank,
            "eps": cfg.eps, "scale": m.scale, "window": m.window, "cache_window": cache_window[i],
            "own_latent": m.kv_from is None, "sinks": True})
        ffn, norms = None, {"norm1": norm("norm1")}
        if layer.mlp is not None:
            f = layer.mlp
            norms["norm2"] = norm("norm2")
            if f.kind == "dense":
                ffn = PartSpec("squared_relu_mlp", {"hidden_size": cfg.width, "intermediate_size": f.ff})
            else:
                shared = None
                if f.shared_ff is not None:
                    shared = PartSpec("clamped_gated_mlp", {"hidden_size": cfg.width, "intermediate_size": f.shared_ff,
                                                            "limit": f.shared_limit, "slope": EXPERT_GATE_SLOPE,
                                                            "up_offset": EXPERT_UP_OFFSET})
                ffn = PartSpec("routed_experts", {"hidden_size": cfg.width, "intermediate_size": f.ff, "experts": f.experts,
                                                  "top": f.top, "limit": f.limit, "slope": EXPERT_GATE_SLOPE,
                                                  "up_offset": EXPERT_UP_OFFSET, "router_bias": True, "shared": shared})
        layers.append(LayerSpec(block="pre_norm", mixer=mixer, ffn=ffn, norms=norms,
                                prefixes={"mixer": "mix.", "ffn": "mlp.", "norm1": "", "norm2": ""},
                                block_params={"residual_scale": cfg.residual_mult}))
        schedule.append(LayerCall(i, cache_of=m.kv_from))
    return ModelSpec(
        architecture="Baselix", vocab_size=cfg.vocab, hidden_size=cfg.width, layers=tuple(layers), schedule=tuple(schedule),
        final_norm=norm("norm"), tie_word_embeddings=True, max_position_embeddings=cfg.max_positions,
        layer_prefix="l{i}.", embed_name="embed", final_norm_prefix="final.", head_name="head",
        embedding=PartSpec("learned_position_embedding", {"vocab_size": cfg.vocab, "hidden_size": cfg.width,
                                                          "max_positions": cfg.max_positions, "name": "embed",
                                                          "position_name": "pos"}),
        head=PartSpec("output_head", {"vocab_size": cfg.vocab, "hidden_size": cfg.width, "tied": True, "name": "head",
                                      "softcap": cfg.logit_softcap}))


BASELIX = register_architecture("Baselix", model_types=("baselix",), parse=parse_baselix_config, build_spec=build_baselix_spec,
                                kernel_libraries=("rowwise", "moe"))
