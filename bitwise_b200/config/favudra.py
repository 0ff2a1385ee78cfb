"""Typed configuration of the Favudra design, read from config.json.

Keys: ``architecture`` ("Favudra"), ``vocab``, ``width``, ``norm.eps``, ``embedding.scale``,
``logit_scale`` and ``layers``, a list with one entry per layer: ``type`` (``attention``,
``attention_2`` or ``gla``), ``mixer`` and ``mlp`` (null for none, else ``kind`` "dense" with
``ff``).  A mixer's keys by type:

* ``attention``: ``heads``, ``kv_heads``, ``dim``, ``vdim``, ``scale``, and optionally ``conv``
  (taps of the short convolution on q, k and v), ``rot.base`` / ``rot.dims``, ``softcap``,
  ``kv_from`` (the layer whose keys and values this one reads);
* ``attention_2``: ``heads``, ``kv_heads``, ``dim``, ``vdim`` (the values are the keys, so it
  equals ``dim``), ``scale``, and optionally ``mask.size`` (the window);
* ``gla``: ``heads``, ``dim``, ``vdim``, ``tau``.

Every size and constant of a model comes from here or from a tensor's shape.
"""
from __future__ import annotations

from dataclasses import dataclass, replace
from typing import Optional, Tuple

from .base import ConfigError

MIXER_TYPES = ("attention", "attention_2", "gla")


def _get(d: dict, key: str, where: str):
    if not isinstance(d, dict) or key not in d:
        raise ConfigError(f"config.json: {where} lacks the key {key!r}")
    return d[key]


def _positive_int(v, what: str) -> int:
    if not isinstance(v, int) or isinstance(v, bool) or v <= 0:
        raise ConfigError(f"config.json: {what} must be a positive integer, got {v!r}")
    return v


def _optional_positive(d: dict, key: str, where: str, kind=int):
    v = d.get(key)
    if v is None:
        return None
    if kind is int:
        return _positive_int(v, f"{where}.{key}")
    v = float(v)
    if not v > 0:
        raise ConfigError(f"config.json: {where}.{key} must be positive, got {v!r}")
    return v


@dataclass(frozen=True)
class FavudraMixerConfig:
    kind: str                        # one of MIXER_TYPES
    heads: int
    dim: int                         # query/key size per head
    vdim: int                        # value size per head
    kv_heads: Optional[int] = None   # the attentions; None for gla
    scale: Optional[float] = None    # the attentions' score scale
    conv: Optional[int] = None       # attention: taps of the short convolution
    rot_base: Optional[float] = None
    rot_dims: Optional[int] = None   # attention: how many leading entries of a head turn
    softcap: Optional[float] = None
    kv_from: Optional[int] = None
    window: Optional[int] = None     # attention_2: keys a position sees, itself included
    tau: Optional[float] = None      # gla: the decay's root
    decay_rank: Optional[int] = None  # gla: inner size of the decay's projection; a tensor's shape, no key of config.json

    @staticmethod
    def from_json(kind: str, d: dict, where: str) -> "FavudraMixerConfig":
        if kind not in MIXER_TYPES:
            raise ConfigError(f"config.json: {where} has the unknown type {kind!r} (known: {', '.join(MIXER_TYPES)})")
        common = dict(kind=kind, heads=_positive_int(_get(d, "heads", where), where + ".heads"),
                      dim=_positive_int(_get(d, "dim", where), where + ".dim"),
                      vdim=_positive_int(_get(d, "vdim", where), where + ".vdim"))
        if kind == "gla":
            tau = float(_get(d, "tau", where))
            if not tau > 0:
                raise ConfigError(f"config.json: {where}.tau must be positive, got {tau!r}")
            return FavudraMixerConfig(tau=tau, **common)
        common.update(kv_heads=_positive_int(_get(d, "kv_heads", where), where + ".kv_heads"),
                      scale=float(_get(d, "scale", where)))
        if common["heads"] % common["kv_heads"]:
            raise ConfigError(f"config.json: {where}: {common['heads']} heads are no multiple of "
                              f"{common['kv_heads']} key/value heads")
        if kind == "attention_2":
            if common["vdim"] != common["dim"]:
                raise ConfigError(f"config.json: {where}: the values are the keys, so vdim must equal dim")
            return FavudraMixerConfig(window=_optional_positive(d.get("mask") or {}, "size", where + ".mask"), **common)
        rot = d.get("rot")
        c = FavudraMixerConfig(conv=_optional_positive(d, "conv", where),
                               rot_base=float(_get(rot, "base", where + ".rot")) if rot else None,
                               rot_dims=_positive_int(_get(rot, "dims", where + ".rot"), where + ".rot.dims") if rot else None,
                               softcap=_optional_positive(d, "softcap", where, float),
                               kv_from=int(d["kv_from"]) if d.get("kv_from") is not None else None, **common)
        if c.rot_dims is not None and (c.rot_dims > c.dim or c.rot_dims % 2):
            raise ConfigError(f"config.json: {where}.rot.dims = {c.rot_dims} must be even and at most dim = {c.dim}")
        if c.rot_base is not None and not c.rot_base > 0:
            raise ConfigError(f"config.json: {where}.rot.base must be positive")
        return c

    def cache_signature(self):
        """What two attention layers must agree on to share keys and values."""
        return (self.kv_heads, self.dim, self.vdim, self.rot_base, self.rot_dims)

    def to_json(self) -> dict:
        d = {"dim": self.dim, "heads": self.heads, "vdim": self.vdim}
        if self.kind == "gla":
            d["tau"] = self.tau
            return d
        d.update(kv_heads=self.kv_heads, scale=self.scale)
        if self.kind == "attention_2":
            if self.window is not None:
                d["mask"] = {"size": self.window}
            return d
        if self.conv is not None:
            d["conv"] = self.conv
        if self.rot_dims is not None:
            d["rot"] = {"base": self.rot_base, "dims": self.rot_dims}
        if self.softcap is not None:
            d["softcap"] = self.softcap
        if self.kv_from is not None:
            d["kv_from"] = self.kv_from
        return d


@dataclass(frozen=True)
class FavudraLayerConfig:
    mixer: FavudraMixerConfig
    ff: Optional[int] = None   # inner size of the dense feed-forward; None: the layer has none


@dataclass(frozen=True)
class FavudraConfig:
    vocab: int
    width: int
    eps: float
    embedding_scale: float
    logit_scale: float
    layers: Tuple[FavudraLayerConfig, ...]
    architectures: tuple = ("Favudra",)
    eos_token_id: int = -1

    architecture_name = "Favudra"

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
                raise ConfigError(f"config.json: layer {i} reads the keys of layer {j}, which is not an earlier layer")
            a, b = self.layers[j].mixer, layer.mixer
            if a.kind != "attention" or a.kv_from is not None:
                raise ConfigError(f"config.json: layer {i} reads the keys of layer {j}, which has none of its own")
            if a.cache_signature() != b.cache_signature():
                raise ConfigError(f"config.json: layers {i} and {j} share keys and differ in head counts, sizes or rotation")

    @property
    def vocab_size(self) -> int:
        return self.vocab

    def with_tensor_shapes(self, shapes) -> "FavudraConfig":
        """The sizes that only a checkpoint's tensors give (name -> shape): the inner size of every
        gla layer's decay projection is the row count of ``l<i>.mix.a1``."""
        layers = []
        for i, layer in enumerate(self.layers):
            shape = shapes.get(f"l{i}.mix.a1")
            if layer.mixer.kind == "gla" and shape is not None and len(shape) == 2:
                layer = replace(layer, mixer=replace(layer.mixer, decay_rank=int(shape[0])))
            layers.append(layer)
        return replace(self, layers=tuple(layers))

    @staticmethod
    def from_json(d: dict) -> "FavudraConfig":
        layers = []
        for i, entry in enumerate(_get(d, "layers", "the model")):
            where = f"layers[{i}]"
            mixer = FavudraMixerConfig.from_json(_get(entry, "type", where), _get(entry, "mixer", where), where + ".mixer")
            mlp = entry.get("mlp")
            ff = None
            if mlp:
                if mlp.get("kind", "dense") != "dense":
                    raise ConfigError(f"config.json: {where}.mlp.kind = {mlp.get('kind')!r} is not supported (supported: 'dense')")
                ff = _positive_int(_get(mlp, "ff", where + ".mlp"), where + ".mlp.ff")
            layers.append(FavudraLayerConfig(mixer, ff))
        eos = d.get("eos_token_id", -1)
        return FavudraConfig(vocab=_get(d, "vocab", "the model"), width=_get(d, "width", "the model"),
                             eps=float(_get(_get(d, "norm", "the model"), "eps", "norm")),
                             embedding_scale=float((d.get("embedding") or {}).get("scale", 1.0)),
                             logit_scale=float(d.get("logit_scale", 1.0)), layers=tuple(layers),
                             eos_token_id=-1 if eos is None else int(eos))

    def to_json(self) -> dict:
        return {"architecture": "Favudra", "embedding": {"scale": self.embedding_scale},
                "layers": [{"mixer": l.mixer.to_json(), "mlp": {"ff": l.ff, "kind": "dense"} if l.ff else None,
                            "type": l.mixer.kind} for l in self.layers],
                "logit_scale": self.logit_scale, "norm": {"eps": self.eps}, "vocab": self.vocab, "width": self.width}
