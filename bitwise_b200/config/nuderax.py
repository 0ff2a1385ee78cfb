"""Typed configuration of the Nuderax design, read from config.json.

Keys: ``architecture`` ("Nuderax"), ``vocab``, ``width``, ``norm.eps`` and ``layers``, a list
with one entry per layer: ``type`` (``latent_attention``: queries straight from the input;
``latent_attention_2``: queries through a latent of ``q_rank`` numbers), ``mixer`` (``heads``,
``dim``, ``rot_dim``, ``vdim``, ``kv_rank``, ``scale``, ``rot.base``, ``rot.dims``, and optionally
``q_rank``, ``kv_from``: the layer whose cache this one reads) and ``mlp`` (null for none, else
``kind`` "moe" with ``router.experts``, ``router.top``, ``router.scale``, ``router.groups.count``,
``router.groups.keep``, ``expert.ff``, ``expert.limit`` and optionally ``shared.ff``,
``shared.limit``).  Every size and constant of a model comes from here or from a tensor's shape.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional, Tuple

from .base import ConfigError

MIXER_TYPES = ("latent_attention", "latent_attention_2")


def _get(d: dict, key: str, where: str):
    if not isinstance(d, dict) or key not in d:
        raise ConfigError(f"config.json: {where} lacks the key {key!r}")
    return d[key]


def _positive_int(v, what: str) -> int:
    if not isinstance(v, int) or isinstance(v, bool) or v <= 0:
        raise ConfigError(f"config.json: {what} must be a positive integer, got {v!r}")
    return v


@dataclass(frozen=True)
class LatentMixerConfig:
    kind: str                 # one of MIXER_TYPES
    heads: int
    dim: int                  # unrotated query/key size per head
    rot_dim: int              # rotated query/key size per head (the key part is shared by the heads)
    vdim: int
    kv_rank: int
    scale: float
    rot_base: float
    rot_dims: int             # how many of the rot_dim entries turn
    q_rank: Optional[int] = None
    kv_from: Optional[int] = None

    @staticmethod
    def from_json(kind: str, d: dict, where: str) -> "LatentMixerConfig":
        if kind not in MIXER_TYPES:
            raise ConfigError(f"config.json: {where} has the unknown type {kind!r} (known: {', '.join(MIXER_TYPES)})")
        rot = _get(d, "rot", where + ".mixer")
        c = LatentMixerConfig(
            kind=kind,
            heads=_positive_int(_get(d, "heads", where), where + ".heads"),
            dim=_positive_int(_get(d, "dim", where), where + ".dim"),
            rot_dim=_positive_int(_get(d, "rot_dim", where), where + ".rot_dim"),
            vdim=_positive_int(_get(d, "vdim", where), where + ".vdim"),
            kv_rank=_positive_int(_get(d, "kv_rank", where), where + ".kv_rank"),
            scale=float(_get(d, "scale", where)),
            rot_base=float(_get(rot, "base", where + ".rot")),
            rot_dims=_positive_int(_get(rot, "dims", where + ".rot"), where + ".rot.dims"),
            q_rank=_positive_int(d["q_rank"], where + ".q_rank") if d.get("q_rank") is not None else None,
            kv_from=int(d["kv_from"]) if d.get("kv_from") is not None else None)
        if c.rot_dims > c.rot_dim or c.rot_dims % 2:
            raise ConfigError(f"config.json: {where}.rot.dims = {c.rot_dims} must be even and at most rot_dim = {c.rot_dim}")
        if not c.rot_base > 0:
            raise ConfigError(f"config.json: {where}.rot.base must be positive")
        if kind == "latent_attention_2" and c.q_rank is None:
            raise ConfigError(f"config.json: {where} is of type latent_attention_2 and lacks q_rank")
        return c

    def to_json(self) -> dict:
        d = {"dim": self.dim, "heads": self.heads, "kv_rank": self.kv_rank,
             "rot": {"base": self.rot_base, "dims": self.rot_dims}, "rot_dim": self.rot_dim, "scale": self.scale,
             "vdim": self.vdim}
        if self.kind == "latent_attention_2":
            d["q_rank"] = self.q_rank
        if self.kv_from is not None:
            d["kv_from"] = self.kv_from
        return d


@dataclass(frozen=True)
class RoutedMlpConfig:
    experts: int
    top: int
    weight_scale: float
    groups: int
    keep_groups: int
    ff: int
    limit: float
    shared_ff: Optional[int] = None
    shared_limit: Optional[float] = None

    @staticmethod
    def from_json(d: dict, where: str) -> "RoutedMlpConfig":
        kind = d.get("kind", "moe")
        if kind != "moe":
            raise ConfigError(f"config.json: {where}.kind = {kind!r} is not supported (supported: 'moe')")
        r = _get(d, "router", where)
        e = _get(d, "expert", where)
        g = r.get("groups") or {"count": 1, "keep": 1}
        shared = d.get("shared")
        c = RoutedMlpConfig(
            experts=_positive_int(_get(r, "experts", where + ".router"), where + ".router.experts"),
            top=_positive_int(_get(r, "top", where + ".router"), where + ".router.top"),
            weight_scale=float(r.get("scale", 1.0)),
            groups=_positive_int(_get(g, "count", where + ".router.groups"), where + ".router.groups.count"),
            keep_groups=_positive_int(_get(g, "keep", where + ".router.groups"), where + ".router.groups.keep"),
            ff=_positive_int(_get(e, "ff", where + ".expert"), where + ".expert.ff"),
            limit=float(_get(e, "limit", where + ".expert")),
            shared_ff=_positive_int(_get(shared, "ff", where + ".shared"), where + ".shared.ff") if shared else None,
            shared_limit=float(_get(shared, "limit", where + ".shared")) if shared else None)
        if c.experts % c.groups:
            raise ConfigError(f"config.json: {where}: {c.experts} experts do not form {c.groups} equal groups")
        if c.keep_groups > c.groups or c.top > c.keep_groups * (c.experts // c.groups):
            raise ConfigError(f"config.json: {where}: {c.top} choices do not fit {c.keep_groups} of {c.groups} groups")
        return c

    def to_json(self) -> dict:
        d = {"expert": {"ff": self.ff, "limit": self.limit}, "kind": "moe",
             "router": {"experts": self.experts, "groups": {"count": self.groups, "keep": self.keep_groups},
                        "scale": self.weight_scale, "top": self.top}}
        if self.shared_ff is not None:
            d["shared"] = {"ff": self.shared_ff, "limit": self.shared_limit}
        return d


@dataclass(frozen=True)
class NuderaxLayerConfig:
    mixer: LatentMixerConfig
    mlp: Optional[RoutedMlpConfig]


@dataclass(frozen=True)
class NuderaxConfig:
    vocab: int
    width: int
    eps: float
    layers: Tuple[NuderaxLayerConfig, ...]
    architectures: tuple = ("Nuderax",)
    eos_token_id: int = -1

    architecture_name = "Nuderax"

    def __post_init__(self):
        _positive_int(self.vocab, "vocab")
        _positive_int(self.width, "width")
        if not self.eps > 0:
            raise ConfigError(f"config.json: norm.eps must be positive, got {self.eps!r}")
        if not self.layers:
            raise ConfigError("config.json: no layers")
        for i, layer in enumerate(self.layers):
            j = layer.mixer.kv_from
            if j is None:
                continue
            if not (0 <= j < i):
                raise ConfigError(f"config.json: layer {i} reads the cache of layer {j}, which is not an earlier layer")
            a, b = self.layers[j].mixer, layer.mixer
            if a.kv_from is not None:
                raise ConfigError(f"config.json: layer {i} reads the cache of layer {j}, which has none of its own")
            if (a.kv_rank, a.rot_dim, a.rot_base, a.rot_dims) != (b.kv_rank, b.rot_dim, b.rot_base, b.rot_dims):
                raise ConfigError(f"config.json: layers {i} and {j} share a cache and differ in its sizes or rotation")

    @property
    def vocab_size(self) -> int:
        return self.vocab

    @staticmethod
    def from_json(d: dict) -> "NuderaxConfig":
        layers = []
        for i, entry in enumerate(_get(d, "layers", "the model")):
            where = f"layers[{i}]"
            mixer = LatentMixerConfig.from_json(_get(entry, "type", where), _get(entry, "mixer", where), where + ".mixer")
            mlp = entry.get("mlp")
            layers.append(NuderaxLayerConfig(mixer, RoutedMlpConfig.from_json(mlp, where + ".mlp") if mlp else None))
        eos = d.get("eos_token_id", -1)
        return NuderaxConfig(vocab=_get(d, "vocab", "the model"), width=_get(d, "width", "the model"),
                             eps=float(_get(_get(d, "norm", "the model"), "eps", "norm")), layers=tuple(layers),
                             eos_token_id=-1 if eos is None else int(eos))

    def to_json(self) -> dict:
        return {"architecture": "Nuderax",
                "layers": [{"mixer": l.mixer.to_json(), "mlp": l.mlp.to_json() if l.mlp else None, "type": l.mixer.kind}
                           for l in self.layers],
                "norm": {"eps": self.eps}, "vocab": self.vocab, "width": self.width}
