"""Typed configuration of the Potuzen design: a decoder whose layers are listed one by one in config.json,
each with its kind of mixer (latent attention behind a sliding window, a state-space mixer, gated linear
attention), the mixer's sizes, and its feed-forward (or none).

config.json keys: `architecture` ("Potuzen"), `vocab`, `width`, `norm.eps`, and `layers`: a list of
`{"type", "mixer": {...}, "mlp": {"kind", "ff"} | null, "weights_of": j (optional)}`.  A layer with
`weights_of` owns no tensors: it runs with layer j's, on a cache or state of its own.
"""
from __future__ import annotations

import dataclasses
from dataclasses import dataclass
from typing import Any, Dict, Mapping, Optional, Tuple

from .llama import ConfigError

ARCHITECTURE = "Potuzen"

# for each kind of mixer: the keys of its `mixer` entry, with the type each is read as
MIXER_KEYS = {
    "latent_attention": {"heads": int, "dim": int, "vdim": int, "kv_rank": int, "q_rank": int, "scale": float, "mask": dict},
    "mamba2": {"heads": int, "vdim": int, "state": int, "groups": int, "conv": int, "norm_groups": int},
    "gla": {"heads": int, "dim": int, "vdim": int, "tau": float},
}
MLP_KINDS = ("dense",)


def _need(d: Mapping[str, Any], key: str, where: str):
    if key not in d:
        raise ConfigError(f"config.json: {where} lacks the key {key!r}")
    return d[key]


@dataclass(frozen=True)
class PotuzenLayer:
    type: str
    mixer: Mapping[str, Any]
    mlp: Optional[Mapping[str, Any]]
    weights_of: Optional[int] = None

    def to_dict(self) -> Dict[str, Any]:
        out: Dict[str, Any] = {"type": self.type, "mixer": _plain(self.mixer), "mlp": _plain(self.mlp)}
        if self.weights_of is not None:
            out["weights_of"] = self.weights_of
        return out


def _plain(v):
    if isinstance(v, Mapping):
        return {k: _plain(x) for k, x in v.items()}
    return v


@dataclass(frozen=True)
class PotuzenConfig:
    vocab: int
    width: int
    norm_eps: float
    layers: Tuple[PotuzenLayer, ...]
    architecture: str = ARCHITECTURE

    @staticmethod
    def from_dict(raw: Mapping[str, Any]) -> "PotuzenConfig":
        vocab, width = int(_need(raw, "vocab", "the model")), int(_need(raw, "width", "the model"))
        eps = float(_need(_need(raw, "norm", "the model"), "eps", "norm"))
        entries = _need(raw, "layers", "the model")
        if not isinstance(entries, (list, tuple)) or not entries:
            raise ConfigError("config.json: 'layers' must be a list with at least one layer")
        if vocab <= 0 or width <= 0 or eps < 0:
            raise ConfigError("config.json: 'vocab' and 'width' must be positive and 'norm.eps' not negative")
        layers = []
        for i, e in enumerate(entries):
            where = f"layers[{i}]"
            kind = _need(e, "type", where)
            if kind not in MIXER_KEYS:
                raise ConfigError(f"config.json: {where}.type={kind!r} is not known ({', '.join(sorted(MIXER_KEYS))})")
            m = _need(e, "mixer", where)
            mixer: Dict[str, Any] = {}
            for key, typ in MIXER_KEYS[kind].items():
                val = _need(m, key, f"{where}.mixer")
                mixer[key] = dict(val) if typ is dict else typ(val)
            if kind == "latent_attention":
                size = int(_need(mixer["mask"], "size", f"{where}.mixer.mask"))
                if size <= 0:
                    raise ConfigError(f"config.json: {where}.mixer.mask.size must be positive")
                mixer["mask"] = {"size": size}
            for key, val in mixer.items():
                if isinstance(val, int) and val <= 0:
                    raise ConfigError(f"config.json: {where}.mixer.{key} must be positive")
            if kind == "mamba2":
                if mixer["heads"] % mixer["groups"]:
                    raise ConfigError(f"config.json: {where}.mixer.heads is not a multiple of groups")
                if (mixer["heads"] * mixer["vdim"]) % mixer["norm_groups"]:
                    raise ConfigError(f"config.json: {where}.mixer: heads * vdim is not a multiple of norm_groups")
            if kind == "gla" and m.get("decay_rank") is not None:
                mixer["decay_rank"] = int(m["decay_rank"])        # optional: the tensors' shapes give it otherwise
            if kind == "gla" and mixer["tau"] <= 0:
                raise ConfigError(f"config.json: {where}.mixer.tau must be positive")
            mlp = e.get("mlp")
            if mlp is not None:
                mk = _need(mlp, "kind", f"{where}.mlp")
                if mk not in MLP_KINDS:
                    raise ConfigError(f"config.json: {where}.mlp.kind={mk!r} is not known ({', '.join(MLP_KINDS)})")
                ff = int(_need(mlp, "ff", f"{where}.mlp"))
                if ff <= 0:
                    raise ConfigError(f"config.json: {where}.mlp.ff must be positive")
                mlp = {"kind": mk, "ff": ff}
            wo = e.get("weights_of")
            layers.append(PotuzenLayer(kind, mixer, mlp, None if wo is None else int(wo)))
        for i, layer in enumerate(layers):
            j = layer.weights_of
            if j is None:
                continue
            if not 0 <= j < len(layers) or j == i or layers[j].weights_of is not None:
                raise ConfigError(f"config.json: layers[{i}].weights_of={j} does not name another layer with tensors of its own")
            o = layers[j]
            if (o.type, _plain(o.mixer), _plain(o.mlp)) != (layer.type, _plain(layer.mixer), _plain(layer.mlp)):
                raise ConfigError(f"config.json: layers[{i}] uses the weights of layers[{j}] but differs from it")
        return PotuzenConfig(vocab, width, eps, tuple(layers))

    def to_dict(self) -> Dict[str, Any]:
        return {"architecture": self.architecture, "vocab": self.vocab, "width": self.width,
                "norm": {"eps": self.norm_eps}, "layers": [layer.to_dict() for layer in self.layers]}

    def replace(self, **kw) -> "PotuzenConfig":
        return dataclasses.replace(self, **kw)
