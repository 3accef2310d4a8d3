"""Typed configuration of the Barovik decoder, read from config.json, and the layers it is made of.

A Barovik model is a list of layers, each with its own sizes: `layers[i]` names the mixer's `type` ("attention": no
rotation, scores capped, chunks of positions, a sink per head, values blended with the first blending layer's; or
"mamba2": a state-space layer) with its sizes under `mixer`, and the feed-forward under `mlp` (`kind` "dense": gated
with the tanh form of GELU; "moe": routed SiLU-gated experts with a shared one; or null: none).  The embedding is
multiplied by `embedding.scale`; every norm is an RMS norm with `norm.eps`; the head is a matrix of its own.
Nothing about the model lives in code: another model of the design has other sizes, counts, constants and another
order of layers.

Tensors: "embed", "l<i>.norm1", "l<i>.norm2", "l<i>.mix.*", "l<i>.mlp.*", "final.norm", "head".
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Mapping, Optional, Tuple

from ..parts.spec import LayerSpec, ModelSpec, PartSpec, ScheduleEntry
from .errors import ConfigError

ARCHITECTURE = "Barovik"
# the design has no position encoding, so no length it was trained for; a cache's default per-sequence limit
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
class AttentionMixer:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    softcap: Optional[float]
    chunk: Optional[int]
    v_mix: bool


@dataclass(frozen=True)
class Mamba2Mixer:
    heads: int
    vdim: int
    state: int
    groups: int
    conv: int
    norm_groups: int


@dataclass(frozen=True)
class DenseMlp:
    ff: int


@dataclass(frozen=True)
class MoeMlp:
    experts: int
    top: int
    expert_ff: int
    shared_ff: Optional[int]


@dataclass(frozen=True)
class BarovikLayer:
    type: str
    mixer: Any
    mlp: Any


@dataclass(frozen=True)
class BarovikConfig:
    architecture: str
    width: int
    vocab: int
    embedding_scale: float
    norm_eps: float
    layers: Tuple[BarovikLayer, ...]
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
        return NO_POSITION_LIMIT

    @property
    def eos_token_ids(self) -> Tuple[int, ...]:
        return self.stop_token_ids

    @classmethod
    def from_dict(cls, raw: Mapping[str, Any]) -> "BarovikConfig":
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
            if kind == "attention":
                heads, kv = _int(m, "heads", where), _int(m, "kv_heads", where)
                if heads % kv:
                    raise ConfigError(f"config.json of {ARCHITECTURE}: {where}: {heads} heads do not divide into {kv} kv heads")
                mask = m.get("mask")
                chunk = _int(mask, "size", where + ".mask") if mask else None
                cap = m.get("softcap")
                mixer = AttentionMixer(heads, kv, _int(m, "dim", where), _int(m, "vdim", where), _num(m, "scale", where),
                                       _num(m, "softcap", where) if cap else None, chunk, bool(m.get("v_mix", False)))
            elif kind == "mamba2":
                heads, groups = _int(m, "heads", where), _int(m, "groups", where)
                if heads % groups:
                    raise ConfigError(f"config.json of {ARCHITECTURE}: {where}: {heads} heads do not divide into {groups} groups")
                mixer = Mamba2Mixer(heads, _int(m, "vdim", where), _int(m, "state", where), groups, _int(m, "conv", where),
                                    _int(m, "norm_groups", where))
                if (mixer.heads * mixer.vdim) % mixer.norm_groups:
                    raise ConfigError(f"config.json of {ARCHITECTURE}: {where}: {mixer.heads * mixer.vdim} values do not "
                                      f"divide into {mixer.norm_groups} norm groups")
            else:
                raise ConfigError(f"config.json of {ARCHITECTURE}: {where}: unknown layer type {kind!r} (attention, mamba2)")
            mr = lr.get("mlp") if isinstance(lr, Mapping) else None
            if mr is None:
                mlp = None
            elif _need(mr, "kind", where + ".mlp") == "dense":
                mlp = DenseMlp(_int(mr, "ff", where + ".mlp"))
            elif mr["kind"] == "moe":
                router = _need(mr, "router", where + ".mlp")
                experts, top = _int(router, "experts", where + ".mlp.router"), _int(router, "top", where + ".mlp.router")
                if top > experts:
                    raise ConfigError(f"config.json of {ARCHITECTURE}: {where}: {top} of {experts} experts cannot be chosen")
                shared = mr.get("shared")
                mlp = MoeMlp(experts, top, _int(_need(mr, "expert", where + ".mlp"), "ff", where + ".mlp.expert"),
                             _int(shared, "ff", where + ".mlp.shared") if shared else None)
            else:
                raise ConfigError(f"config.json of {ARCHITECTURE}: {where}: unknown feed-forward kind {mr['kind']!r} (dense, moe)")
            layers.append(BarovikLayer(kind, mixer, mlp))
        stops = raw.get("eos_token_id")
        stops = () if stops is None else tuple(int(t) for t in (stops if isinstance(stops, (list, tuple)) else [stops]))
        return cls(ARCHITECTURE, width, vocab, _num(_need(raw, "embedding", "the top level"), "scale", "embedding"),
                   _num(_need(raw, "norm", "the top level"), "eps", "norm"), tuple(layers), stops)


def build_barovik_spec(cfg: BarovikConfig) -> ModelSpec:
    bare = {"tensor_names": {"weight": ""}}      # "l0.norm1", "embed", "head": the tensor is the prefix itself
    norm = PartSpec("rmsnorm", {"size": cfg.width, "eps": cfg.norm_eps, **bare})
    layers = []
    ignorable = []          # tensors a file may hold for what this model's configuration switches off
    seen_blend = False
    for i, layer in enumerate(cfg.layers):
        m = layer.mixer
        if layer.mlp is None:
            ignorable.append(f"l{i}.norm2")
        if layer.type == "attention":
            role = None
            if m.v_mix:
                role, seen_blend = ("blend" if seen_blend else "source"), True
            else:
                ignorable.append(f"l{i}.mix.vmix")
            mixer = PartSpec("sink_attention", {
                "hidden_size": cfg.width, "num_heads": m.heads, "num_kv_heads": m.kv_heads, "head_dim": m.dim,
                "v_head_dim": m.vdim, "scale": m.scale, "softcap": m.softcap, "sink": True, "chunk": m.chunk,
                "window": None, "value_mix": role, "value_mix_key": "barovik_first_values"})
        else:
            mixer = PartSpec("mamba2", {
                "hidden_size": cfg.width, "heads": m.heads, "head_dim": m.vdim, "state": m.state, "groups": m.groups,
                "conv": m.conv, "norm_groups": m.norm_groups, "eps": cfg.norm_eps})
        if layer.mlp is None:
            ffn = None
        elif isinstance(layer.mlp, DenseMlp):
            ffn = PartSpec("gated_mlp", {"hidden_size": cfg.width, "intermediate_size": layer.mlp.ff, "activation": "gelu_tanh",
                                         "tensor_names": {"gate": "mlp.gate", "up": "mlp.up", "down": "mlp.down"}})
        else:
            ffn = PartSpec("routed_experts", {"hidden_size": cfg.width, "experts": layer.mlp.experts, "top": layer.mlp.top,
                                              "expert_ff": layer.mlp.expert_ff, "shared_ff": layer.mlp.shared_ff})
        layers.append(LayerSpec(prefix=f"l{i}.", block="prenorm_residual", mixer_norm=norm, mixer=mixer,
                                ffn_norm=norm if ffn is not None else None, ffn=ffn,
                                mixer_norm_prefix="norm1", ffn_norm_prefix="norm2"))
    spec = ModelSpec(
        architecture=cfg.architecture, hidden_size=cfg.width, vocab_size=cfg.vocab, max_positions=NO_POSITION_LIMIT,
        embedding=PartSpec("token_embedding", {"vocab_size": cfg.vocab, "hidden_size": cfg.width, "scale": cfg.embedding_scale, **bare}),
        layers=tuple(layers), schedule=tuple(ScheduleEntry(i) for i in range(len(layers))), final_norm=norm,
        head=PartSpec("linear_head", {"vocab_size": cfg.vocab, "hidden_size": cfg.width, "tied": False, **bare}),
        stop_token_ids=cfg.stop_token_ids, embedding_prefix="embed", final_norm_prefix="final.norm", head_prefix="head",
        ignorable_tensors=tuple(ignorable))
    spec.validate()
    return spec
