"""Typed configuration of the Kunulorn design: a decoder whose layers are listed one by one in config.json, each an
attention mixer (biased projections, a norm over the whole of q and of k, a partial rotation in neighbouring pairs, a
mask of chunks, optionally the keys and values of an earlier layer) and a feed-forward that is dense (clamped
branches), routed (a mixture of experts with a shared expert) or absent.

config.json keys: `architecture` ("Kunulorn"), `vocab`, `width`, `norm.eps`, `embedding.scale`, and `layers`: a list
of `{"type": "attention", "mixer": {heads, kv_heads, dim, vdim, scale, mask: {size}, rot: {base, dims}, kv_from?},
"mlp": null | {"kind": "dense", ff, limit} | {"kind": "moe", expert: {ff}, router: {experts, top, scale,
groups?: {count, keep}}, shared?: {ff}}}`.  Every size and constant is read from there; nothing is assumed equal
between layers.
"""
from __future__ import annotations

import dataclasses
from dataclasses import dataclass
from typing import Any, Dict, Mapping, Optional, Tuple

from .llama import ConfigError

ARCHITECTURE = "Kunulorn"
MIXER_TYPES = ("attention",)
MLP_KINDS = ("dense", "moe")


def _need(d: Mapping[str, Any], key: str, where: str):
    if not isinstance(d, Mapping) or key not in d:
        raise ConfigError(f"config.json: {where} lacks the key {key!r}")
    return d[key]


def _positive(v, what: str, kind=int):
    try:
        out = kind(v)
    except (TypeError, ValueError):
        raise ConfigError(f"config.json: {what} must be a number, not {v!r}") from None
    if not out > 0:
        raise ConfigError(f"config.json: {what} must be positive")
    return out


def _plain(v):
    if isinstance(v, Mapping):
        return {k: _plain(x) for k, x in v.items()}
    return v


@dataclass(frozen=True)
class KunulornLayer:
    type: str
    mixer: Mapping[str, Any]            # heads, kv_heads, dim, vdim, scale, mask_size, rot_base, rot_dims, kv_from
    mlp: Optional[Mapping[str, Any]]    # None | {"kind": "dense", ...} | {"kind": "moe", ...}, as in config.json

    def to_dict(self) -> Dict[str, Any]:
        m = self.mixer
        mixer = {"heads": m["heads"], "kv_heads": m["kv_heads"], "dim": m["dim"], "vdim": m["vdim"], "scale": m["scale"]}
        if m["mask_size"] is not None:
            mixer["mask"] = {"size": m["mask_size"]}
        if m["rot_dims"] or m.get("rot_given"):
            mixer["rot"] = {"base": m["rot_base"], "dims": m["rot_dims"]}
        if m.get("kv_from") is not None:
            mixer["kv_from"] = m["kv_from"]
        return {"type": self.type, "mixer": mixer, "mlp": _plain(self.mlp)}


def _read_mixer(m, where: str) -> Dict[str, Any]:
    out = {k: _positive(_need(m, k, where), f"{where}.{k}") for k in ("heads", "kv_heads", "dim", "vdim")}
    out["scale"] = float(_need(m, "scale", where))
    # a mixer without `mask` sees every earlier key; one without `rot` rotates nothing
    out["mask_size"] = None
    if m.get("mask") is not None:
        out["mask_size"] = _positive(_need(m["mask"], "size", where + ".mask"), f"{where}.mask.size")
    out["rot_base"], out["rot_dims"] = 10000.0, 0
    if m.get("rot") is not None:
        rot = m["rot"]
        out["rot_base"] = _positive(_need(rot, "base", where + ".rot"), f"{where}.rot.base", float)
        out["rot_dims"] = int(_need(rot, "dims", where + ".rot"))
    if out["heads"] % out["kv_heads"]:
        raise ConfigError(f"config.json: {where}.heads is not a multiple of kv_heads")
    if out["rot_dims"] < 0 or out["rot_dims"] % 2 or out["rot_dims"] > out["dim"]:
        raise ConfigError(f"config.json: {where}.rot.dims must be even and at most dim")
    out["kv_from"] = None if m.get("kv_from") is None else int(m["kv_from"])
    out["rot_given"] = m.get("rot") is not None
    return out


def _read_mlp(mlp, where: str) -> Optional[Dict[str, Any]]:
    if mlp is None:
        return None
    kind = _need(mlp, "kind", where)
    if kind not in MLP_KINDS:
        raise ConfigError(f"config.json: {where}.kind={kind!r} is not known ({', '.join(MLP_KINDS)})")
    if kind == "dense":
        return {"kind": "dense", "ff": _positive(_need(mlp, "ff", where), f"{where}.ff"),
                "limit": _positive(_need(mlp, "limit", where), f"{where}.limit", float)}
    r = _need(mlp, "router", where)
    router: Dict[str, Any] = {"experts": _positive(_need(r, "experts", where + ".router"), f"{where}.router.experts"),
                              "top": _positive(_need(r, "top", where + ".router"), f"{where}.router.top"),
                              "scale": float(_need(r, "scale", where + ".router"))}
    if router["top"] > router["experts"]:
        raise ConfigError(f"config.json: {where}.router.top exceeds the number of experts")
    if r.get("groups") is not None:
        g = r["groups"]
        count = _positive(_need(g, "count", where + ".router.groups"), f"{where}.router.groups.count")
        keep = _positive(_need(g, "keep", where + ".router.groups"), f"{where}.router.groups.keep")
        if router["experts"] % count or keep > count:
            raise ConfigError(f"config.json: {where}.router.groups: the experts do not form {count} equal groups of which {keep} are kept")
        if router["top"] > keep * (router["experts"] // count):
            raise ConfigError(f"config.json: {where}.router: the kept groups hold fewer experts than 'top'")
        router["groups"] = {"count": count, "keep": keep}
    out: Dict[str, Any] = {"kind": "moe", "router": router,
                           "expert": {"ff": _positive(_need(_need(mlp, "expert", where), "ff", where + ".expert"), f"{where}.expert.ff")}}
    if mlp.get("shared") is not None:
        out["shared"] = {"ff": _positive(_need(mlp["shared"], "ff", where + ".shared"), f"{where}.shared.ff")}
    return out


@dataclass(frozen=True)
class KunulornConfig:
    vocab: int
    width: int
    norm_eps: float
    embedding_scale: float
    layers: Tuple[KunulornLayer, ...]
    architecture: str = ARCHITECTURE

    @staticmethod
    def from_dict(raw: Mapping[str, Any]) -> "KunulornConfig":
        vocab = _positive(_need(raw, "vocab", "the model"), "'vocab'")
        width = _positive(_need(raw, "width", "the model"), "'width'")
        eps = float(_need(_need(raw, "norm", "the model"), "eps", "norm"))
        if eps < 0:
            raise ConfigError("config.json: 'norm.eps' must not be negative")
        scale = float(_need(_need(raw, "embedding", "the model"), "scale", "embedding"))   # (named in full: a model says its scale)
        entries = _need(raw, "layers", "the model")
        if not isinstance(entries, (list, tuple)) or not entries:
            raise ConfigError("config.json: 'layers' must be a list with at least one layer")
        layers = []
        for i, e in enumerate(entries):
            where = f"layers[{i}]"
            kind = _need(e, "type", where)
            if kind not in MIXER_TYPES:
                raise ConfigError(f"config.json: {where}.type={kind!r} is not known ({', '.join(MIXER_TYPES)})")
            m = _need(e, "mixer", where)
            j = m.get("kv_from") if isinstance(m, Mapping) else None
            if isinstance(j, int) and 0 <= j < i and isinstance(entries[j].get("mixer"), Mapping):
                # what a borrowing layer shares with the layer it borrows from may be left out of its entry
                m = dict(m)
                for key in ("kv_heads", "dim", "vdim", "rot"):
                    if key not in m and key in entries[j]["mixer"]:
                        m[key] = entries[j]["mixer"][key]
            layers.append(KunulornLayer(kind, _read_mixer(m, where + ".mixer"), _read_mlp(e.get("mlp"), where + ".mlp")))
        for i, layer in enumerate(layers):
            j = layer.mixer["kv_from"]
            if j is None:
                continue
            if not 0 <= j < i or layers[j].mixer["kv_from"] is not None:
                raise ConfigError(f"config.json: layers[{i}].mixer.kv_from={j} does not name an earlier layer with keys and "
                                  f"values of its own")
            a, b = layer.mixer, layers[j].mixer
            for key in ("kv_heads", "dim", "vdim", "rot_base", "rot_dims"):
                if a[key] != b[key]:
                    raise ConfigError(f"config.json: layers[{i}] uses the keys and values of layers[{j}] but its {key} differs")
        return KunulornConfig(vocab, width, eps, scale, tuple(layers))

    def to_dict(self) -> Dict[str, Any]:
        return {"architecture": self.architecture, "vocab": self.vocab, "width": self.width,
                "norm": {"eps": self.norm_eps}, "embedding": {"scale": self.embedding_scale},
                "layers": [layer.to_dict() for layer in self.layers]}

    def replace(self, **kw) -> "KunulornConfig":
        return dataclasses.replace(self, **kw)
