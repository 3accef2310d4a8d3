"""Typed configuration of the Navalorn decoder, read from config.json, and the layers it is made of.

A Navalorn model is a list of layers.  `layers[i]` names its mixer's `type` ("latent_attention": causal attention whose
keys and values come out of one cached low-rank latent per token, queries through a latent of their own, rotary positions
with YaRN-stretched frequencies on a separate part of queries and keys), the mixer's sizes and constants under `mixer`
(`heads`, `dim`, `rot_dim`, `vdim`, `kv_rank`, `q_rank`, `scale`, `rot` = {`base`, `dims`, `scaling` = {`factor`,
`original`, `fast`, `slow`}}), and the feed-forward under `mlp` (`kind` "dense": W_down relu(W_up h + b)^2 + b, width `ff`;
"moe": `router.experts` ungated experts of width `expert.ff`, of which a token uses `router.top`, weighted on their inputs
by the sigmoids of the router's products; or null: none).  A layer with `weights_of`: j runs layer j's tensors again,
with a cache of its own.  The embedded tokens go through a norm before the first layer; every norm across the width is a
layer norm with a weight and no bias (`norm.eps`); the head is the embedding table.
Nothing about the model lives in code: another model of the design has other sizes, counts, constants and another order
of layers.

Tensors: "embed", "embed.norm", "l<i>.norm1", "l<i>.norm2", "l<i>.mix.*", "l<i>.mlp.*", "final.norm".
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Mapping, Optional, Tuple

from ..parts.spec import LayerSpec, ModelSpec, PartSpec, ScheduleEntry
from .errors import ConfigError

ARCHITECTURE = "Navalorn"
# positions a cache allows per sequence by default where the rotary scaling names no length
NO_POSITION_LIMIT = 1 << 20


def _need(d: Any, key: str, where: str):
    if not isinstance(d, Mapping) or key not in d or d[key] is None:
        raise ConfigError(f"config.json of {ARCHITECTURE}: missing key \"{key}\" in {where}")
    return d[key]


def _int(d: Any, key: str, where: str, least: int = 1) -> int:
    v = _need(d, key, where)
    if isinstance(v, bool) or not isinstance(v, (int, float)) or int(v) != v or int(v) < least:
        raise ConfigError(f"config.json of {ARCHITECTURE}: \"{key}\" in {where} must be an integer >= {least}, got {v!r}")
    return int(v)


def _num(d: Any, key: str, where: str) -> float:
    v = _need(d, key, where)
    if isinstance(v, bool) or not isinstance(v, (int, float)):
        raise ConfigError(f"config.json of {ARCHITECTURE}: \"{key}\" in {where} must be a number, got {v!r}")
    return float(v)


@dataclass(frozen=True)
class RotaryScaling:
    factor: float
    original: float
    fast: float
    slow: float


@dataclass(frozen=True)
class Rotary:
    base: float
    dims: int
    scaling: Optional[RotaryScaling]


@dataclass(frozen=True)
class LatentMixer:
    heads: int
    dim: int
    rot_dim: int
    vdim: int
    kv_rank: int
    q_rank: int
    scale: float
    rot: Optional[Rotary]


@dataclass(frozen=True)
class DenseMlp:
    ff: int


@dataclass(frozen=True)
class MoeMlp:
    experts: int
    top: int
    expert_ff: int


@dataclass(frozen=True)
class NavalornLayer:
    type: str
    mixer: Any
    mlp: Any
    weights_of: Optional[int] = None


def _rotary(m: Any, where: str, rot_dim: int) -> Optional[Rotary]:
    if rot_dim == 0:
        return None
    r = _need(m, "rot", where)
    dims = _int(r, "dims", where + ".rot", least=2)
    if dims % 2 or dims > rot_dim:
        raise ConfigError(f"config.json of {ARCHITECTURE}: {where}.rot: {dims} rotated numbers must be even and at most rot_dim {rot_dim}")
    base = _num(r, "base", where + ".rot")
    if base <= 1.0:
        raise ConfigError(f"config.json of {ARCHITECTURE}: {where}.rot: base must be above 1, got {base}")
    sc = r.get("scaling") if isinstance(r, Mapping) else None
    scaling = None
    if sc:
        w = where + ".rot.scaling"
        scaling = RotaryScaling(_num(sc, "factor", w), _num(sc, "original", w), _num(sc, "fast", w), _num(sc, "slow", w))
        if min(scaling.factor, scaling.original, scaling.fast, scaling.slow) <= 0:
            raise ConfigError(f"config.json of {ARCHITECTURE}: {w}: factor, original, fast and slow must be positive")
    return Rotary(base, dims, scaling)


@dataclass(frozen=True)
class NavalornConfig:
    architecture: str
    width: int
    vocab: int
    norm_eps: float
    layers: Tuple[NavalornLayer, ...]
    stop_token_ids: Tuple[int, ...] = ()

    # what the rest of the library asks of any configuration
    @property
    def vocab_size(self) -> int:
        return self.vocab

    @property
    def hidden_size(self) -> int:
        return self.width

    @property
    def num_hidden_layers(self) -> int:
        return len(self.layers)

    @property
    def max_position_embeddings(self) -> int:
        longest = 0
        for layer in self.layers:
            rot = layer.mixer.rot
            if rot is None or rot.scaling is None:
                return NO_POSITION_LIMIT
            longest = max(longest, int(rot.scaling.original * rot.scaling.factor))
        return longest or NO_POSITION_LIMIT

    @property
    def eos_token_ids(self) -> Tuple[int, ...]:
        return self.stop_token_ids

    @classmethod
    def from_dict(cls, raw: Mapping[str, Any]) -> "NavalornConfig":
        width = _int(raw, "width", "the top level")
        vocab = _int(raw, "vocab", "the top level")
        layers_raw = _need(raw, "layers", "the top level")
        if not isinstance(layers_raw, (list, tuple)) or not layers_raw:
            raise ConfigError(f"config.json of {ARCHITECTURE}: \"layers\" must be a non-empty list")
        layers = []
        for i, lr in enumerate(layers_raw):
            where = f"layers[{i}]"
            kind = _need(lr, "type", where)
            m = _need(lr, "mixer", where)
            if kind != "latent_attention":
                raise ConfigError(f"config.json of {ARCHITECTURE}: {where}: unknown layer type {kind!r} (latent_attention)")
            rot_dim = _int(m, "rot_dim", where, least=0)
            mixer = LatentMixer(_int(m, "heads", where), _int(m, "dim", where), rot_dim, _int(m, "vdim", where),
                                _int(m, "kv_rank", where), _int(m, "q_rank", where), _num(m, "scale", where),
                                _rotary(m, where, rot_dim))
            mr = lr.get("mlp")
            if mr is None:
                mlp = None
            elif _need(mr, "kind", where + ".mlp") == "dense":
                mlp = DenseMlp(_int(mr, "ff", where + ".mlp"))
            elif mr["kind"] == "moe":
                router = _need(mr, "router", where + ".mlp")
                experts, top = _int(router, "experts", where + ".mlp.router"), _int(router, "top", where + ".mlp.router")
                if top > experts:
                    raise ConfigError(f"config.json of {ARCHITECTURE}: {where}: {top} of {experts} experts cannot be chosen")
                mlp = MoeMlp(experts, top, _int(_need(mr, "expert", where + ".mlp"), "ff", where + ".mlp.expert"))
            else:
                raise ConfigError(f"config.json of {ARCHITECTURE}: {where}: unknown feed-forward kind {mr['kind']!r} (dense, moe)")
            src = lr.get("weights_of")
            if src is not None:
                if isinstance(src, bool) or not isinstance(src, int) or not (0 <= src < len(layers_raw)) or src == i:
                    raise ConfigError(f"config.json of {ARCHITECTURE}: {where}: \"weights_of\" must name another layer, got {src!r}")
            layers.append(NavalornLayer(kind, mixer, mlp, src))
        for i, layer in enumerate(layers):
            # a layer that borrows its tensors has the lender's sizes
            j, hops = layer.weights_of, 0
            while j is not None:
                if (layers[j].mixer, layers[j].mlp) != (layer.mixer, layer.mlp):
                    raise ConfigError(f"config.json of {ARCHITECTURE}: layers[{i}] uses the tensors of layers[{j}] but has other sizes")
                j, hops = layers[j].weights_of, hops + 1
                if hops > len(layers):
                    raise ConfigError(f"config.json of {ARCHITECTURE}: \"weights_of\" of layers[{i}] goes round in a circle")
        stops = raw.get("eos_token_id")
        stops = () if stops is None else tuple(int(t) for t in (stops if isinstance(stops, (list, tuple)) else [stops]))
        return cls(ARCHITECTURE, width, vocab, _num(_need(raw, "norm", "the top level"), "eps", "norm"), tuple(layers), stops)


def build_navalorn_spec(cfg: NavalornConfig) -> ModelSpec:
    bare = {"tensor_names": {"weight": ""}}      # "l0.norm1", "embed", "final.norm": the tensor is the prefix itself
    norm = PartSpec("layernorm", {"size": cfg.width, "eps": cfg.norm_eps, **bare})
    layers = []
    spec_of = {}            # index in config.json -> index among the layers that have tensors of their own
    schedule = []
    ignorable = []
    for i, layer in enumerate(cfg.layers):
        src = i
        while cfg.layers[src].weights_of is not None:
            src = cfg.layers[src].weights_of
        if src != i:
            continue
        m = layer.mixer
        position = None
        if m.rot is not None:
            sc = m.rot.scaling
            position = PartSpec("rotary", {
                "head_dim": m.rot_dim, "rotary_dim": m.rot.dims, "theta": m.rot.base, "pairing": "adjacent",
                "scaling": None if sc is None else {"rope_type": "yarn", "factor": sc.factor, "original": sc.original,
                                                    "fast": sc.fast, "slow": sc.slow}})
        mixer = PartSpec("latent_attention", {
            "hidden_size": cfg.width, "num_heads": m.heads, "head_dim": m.dim, "rot_dim": m.rot_dim, "v_head_dim": m.vdim,
            "kv_rank": m.kv_rank, "q_rank": m.q_rank, "scale": m.scale, "eps": cfg.norm_eps, "position": position})
        if layer.mlp is None:
            ffn = None
            ignorable.append(f"l{i}.norm2")
        elif isinstance(layer.mlp, DenseMlp):
            ffn = PartSpec("mlp", {"hidden_size": cfg.width, "intermediate_size": layer.mlp.ff, "activation": "relu2", "bias": True})
        else:
            ffn = PartSpec("scored_experts", {"hidden_size": cfg.width, "experts": layer.mlp.experts, "top": layer.mlp.top,
                                              "expert_ff": layer.mlp.expert_ff, "activation": "relu2", "scores": "sigmoid",
                                              "weight_on": "input"})
        spec_of[i] = len(layers)
        layers.append(LayerSpec(prefix=f"l{i}.", block="prenorm_residual", mixer_norm=norm, mixer=mixer,
                                ffn_norm=norm if ffn is not None else None, ffn=ffn,
                                mixer_norm_prefix="norm1", ffn_norm_prefix="norm2"))
    for i, layer in enumerate(cfg.layers):
        src = i
        while cfg.layers[src].weights_of is not None:
            src = cfg.layers[src].weights_of
        schedule.append(ScheduleEntry(spec_of[src]))          # the same tensors again; every entry keeps a cache of its own
    spec = ModelSpec(
        architecture=cfg.architecture, hidden_size=cfg.width, vocab_size=cfg.vocab, max_positions=cfg.max_position_embeddings,
        embedding=PartSpec("token_embedding", {"vocab_size": cfg.vocab, "hidden_size": cfg.width, **bare}),
        layers=tuple(layers), schedule=tuple(schedule), final_norm=norm,
        head=PartSpec("linear_head", {"vocab_size": cfg.vocab, "hidden_size": cfg.width, "tied": True, **bare}),
        stop_token_ids=cfg.stop_token_ids, embedding_prefix="embed", final_norm_prefix="final.norm", head_prefix="head",
        ignorable_tensors=tuple(ignorable), embedding_norm=norm, embedding_norm_prefix="embed.norm")
    spec.validate()
    return spec
